// The projection as CTA PAIRS: tcgen05.mma.cta_group::2, a 256 x 256 output tile over two SMs of a cluster.
// Included by qkv_gemm.cu (shares its tile constants, Seg / GemmParams, tile decoding and tensor maps).
//
// A single CTA issuing 128 x 256 x 16 MMAs from shared memory reads 12 KiB of operands per instruction and sustains one
// instruction per 167 clocks (3 145 MAC/clk/SM measured).  As a pair each CTA supplies its own 128 rows of x and only
// HALF of the 64 x 256 weight block — 8 KiB per instruction and SM — and the same probe measures 129 clocks (4 068
// MAC/clk/SM).  Every CTA loads its own operands (no multicast): its x tile and its 128 weight columns per k step, a
// stage is 32 KiB and six stages fit.  The leader (rank 0) issues the MMAs for both; barriers:
//   full[stage]   in the LEADER: both CTAs announce their 32 KiB (arrive.expect_tx, the peer remotely) and both CTAs'
//                 TMA loads complete on it
//   empty[stage]  in each CTA: the leader commits the stage's MMAs to its own and to the peer's
//   tfull[acc]    in each CTA: committed likewise when a tile's accumulator is complete (each CTA's TMEM holds its
//                 128 rows x 256 columns, two accumulators)
//   tempty[acc]   in the LEADER: the 2 x 128 epilogue threads of both CTAs arrive (the peer's remotely)
// Bounded waits, status word and teardown as in the single-CTA kernel; the pair meets at hardware cluster barriers
// only (after allocation, before deallocation), which every thread reaches on every path.

constexpr int kG2Threads = 192;
constexpr int kG2BN = 256;
constexpr int kG2Stages = 6;
constexpr int kG2BHalfBytes = 2 * kBBlockBytes;                    // 128 weight columns x 64 k: 16 KiB
constexpr int kG2StageBytes = kABytes + kG2BHalfBytes;             // 32 KiB
constexpr int kG2SmemBytes = kG2Stages * kG2StageBytes + kBarBytes + 1024;

__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem, 128 rows per CTA] * B[smem, half of the columns per CTA]
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// arrives on `bar` (an address of the cluster's shared window: this CTA's or the peer's) when every MMA issued so far
// by this thread has completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// TMA tile load whose completion bytes go to a barrier of the pair's leader (`bar`: cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(m), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kG2Threads, 1)
qkv_gemm2_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w0,
                 const __grid_constant__ CUtensorMap tm_w1, const __grid_constant__ CUtensorMap tm_w2,
                 const __grid_constant__ GemmParams p) {
  constexpr int BN = kG2BN, kStages = kG2Stages, kStageBytes = kG2StageBytes;
  constexpr int kTmemCols = 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kStages * kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* tmem_ptr_smem =
      reinterpret_cast<volatile uint32_t*>(smem_gen + kStages * kStageBytes + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  volatile int* skip_flag = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();           // 0: leader (issues the MMAs), 1: peer
  Ctl ctl{p.status, abort_flag};

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 2);                      // one arrive.expect_tx per CTA (used in the leader only)
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 256);                  // the epilogue threads of both CTAs (used in the leader only)
    }
    *abort_flag = 0;
    // an earlier kernel gave up: do no work, but keep the allocation and the cluster barriers (the two CTAs may read
    // different values of the word; neither may wait for one that left)
    *skip_flag = *reinterpret_cast<volatile int*>(p.status);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                 // both CTAs' barriers are initialised and their TMEM allocated
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const bool active = *skip_flag == 0;
  griddep_wait();
  griddep_launch();

  const int k_steps = (p.K + BK - 1) / BK;
  const int n_pairs = static_cast<int>(gridDim.x) >> 1;
  const int pair = static_cast<int>(blockIdx.x) >> 1;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tm_x);
      tma_prefetch_desc(&tm_w0);
      tma_prefetch_desc(&tm_w1);
      tma_prefetch_desc(&tm_w2);
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = active;
    for (int t = pair; t < p.total_tiles && ok; t += n_pairs) {
      const TileCoord tc = decode_tile(p, t);
      const CUtensorMap* tm_w = tc.seg == 0 ? &tm_w0 : (tc.seg == 1 ? &tm_w1 : &tm_w2);
      for (int ks = 0; ks < k_steps; ++ks) {
        ok = mbar_wait(empty_bar(stage), phase ^ 1u, ctl, KST_TIMEOUT_PRODUCER);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
          const uint32_t lead_full = map_to_rank(full_bar(stage), 0);
          mbar_expect_tx_cluster(lead_full, kStageBytes);
          // this CTA's 128 rows of x and its 128 columns of the 256-column weight block
          tma_load_2d_pair(sa, &tm_x, lead_full, ks * BK, tc.m_tile * (2 * BM) + static_cast<int>(rank) * BM);
#pragma unroll
          for (int c = 0; c < 2; ++c)
            tma_load_2d_pair(sb + c * kBBlockBytes, tm_w, lead_full, tc.n_tile * BN + (static_cast<int>(rank) * 2 + c) * 64,
                             ks * BK);
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader only) -------------------------------
    if (rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(Io<T>::kFmt, /*a_mn=*/0, /*b_mn=*/1, 2 * BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = active;
      int it = 0;
      for (int t = pair; t < p.total_tiles && ok; t += n_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        // a segment's partial last tile: MMAs only as wide as its columns (rounded up to 128: each CTA supplies half)
        uint32_t idesc_t = idesc;
        {
          const TileCoord tcm = decode_tile(p, t);
          const int n_valid = p.seg[tcm.seg].n - tcm.n_tile * BN;
          if (n_valid <= BN / 2) idesc_t = make_idesc_f16(Io<T>::kFmt, /*a_mn=*/0, /*b_mn=*/1, 2 * BM, BN / 2);
        }
        ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, ctl, KST_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int ks = 0; ks < k_steps; ++ks) {
          ok = mbar_wait(full_bar(stage), phase, ctl, KST_TIMEOUT_MMA);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          if (lane == 0) {
            const uint32_t sa = smem_base + stage * kStageBytes;
            const uint32_t sb = sa + kABytes;
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
              const uint64_t adesc = make_smem_desc(sa + kk * 32, 0, 1024);
              const uint64_t bdesc = make_smem_desc(sb + kk * 2048, kBBlockBytes, 1024);
              umma_ss_pair(d_tmem, adesc, bdesc, idesc_t, (ks | kk) != 0 ? 1u : 0u);
            }
            // frees the stage in both CTAs when these MMAs have read it
            umma_commit_pair(empty_bar(stage));
            umma_commit_pair(map_to_rank(empty_bar(stage), 1));
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (lane == 0) {
          umma_commit_pair(tfull_bar(acc));
          umma_commit_pair(map_to_rank(tfull_bar(acc), 1));
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------- epilogue (warps 2..5, both CTAs) -------------------------------
    const int quad = warp & 3;                   // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    const int r_in_tile = quad * 32 + lane;
    const int heads_per_tile = BN / p.D;
    const int chunks_per_head = p.D / 32;
    const float inv_d = 1.0f / static_cast<float>(p.D);
    bool ok = active;
    int it = 0;
    for (int t = pair; t < p.total_tiles && ok; t += n_pairs, ++it) {
      const TileCoord tc = decode_tile(p, t);
      const Seg& sg = p.seg[tc.seg];
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait(tfull_bar(acc), acc_phase, ctl, KST_TIMEOUT_CONSUMER);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();

      const int row = tc.m_tile * (2 * BM) + static_cast<int>(rank) * BM + r_in_tile;
      const bool valid_row = row < p.rows;
      const int b = valid_row ? row / p.rows_per_batch : 0;
      const int s = valid_row ? row - b * p.rows_per_batch : 0;
      const float rscale = (valid_row && p.row_scale != nullptr) ? __ldg(p.row_scale + row) : 1.0f;
      T* out_row = static_cast<T*>(sg.out) + static_cast<long long>(b) * sg.stride_b +
                   static_cast<long long>(sg.row_off + s) * sg.stride_s;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
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
      mbar_arrive_cluster(map_to_rank(tempty_bar(acc), 0));      // the leader's MMA warp waits for both CTAs
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
  tc_fence_before();
  cluster_sync_all();             // neither CTA frees tensor memory (or exits) while the pair's MMAs may still write it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}
