// LoRA linear layer for at most 16 tokens (the reference's lora_benchmark.py shapes: M = 16, N = 1024 / 2048,
// P = 512 / 1024, R = 64 / 128):   d = x a  (stored, 16 bit),   o = x w + d b   (one fp32 sum, rounded once).
//
// At these sizes the operator is one launch of a few microseconds: what counts is latency, not the tensor pipe's
// rate, so this path does without tensor memory, TMA descriptors and a second launch.  A thread-block cluster of up
// to 8 CTAs owns 32 output columns and splits the contraction: warp w of the CTA of rank r contracts the k range
// number 4 r + w of BOTH x w (the cluster's 32 columns) and x a (all R columns, recomputed by every cluster: a comes
// from L2) with warp-level mma.m16n8k16 and fp32 accumulators, streaming its panels of w and a through a private
// cp.async ring (no CTA barrier in the loop).  With 16 or 32 column tiles the split is what puts 128 SMs to work: one
// SM streams ~90 KB per microsecond, and a tile's panels are 192 to 640 KB.  Partial sums are added in a fixed order —
// the four warps of a CTA through its shared memory, then the CTAs in rank order through rank 0's shared memory
// (st.shared::cluster between two cluster barriers) — d is rounded to 16 bit there (cluster 0 stores it), and the
// small product d b is added before the single rounding of o.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "host.h"
#include "small_mma.cuh"

namespace trn {
namespace {

constexpr int kLsThreads = 128;
constexpr int kLsCols = 32;        // output columns per CTA
constexpr int kLsKC = 32;          // k rows per ring stage
constexpr int kLsStages = 3;
constexpr int kLsWPitch = kLsCols + 8;      // 16-bit elements per staged row of w / b: 80 bytes, conflict-free ldmatrix

template <int R>
struct LsSmem {
  static constexpr int kAPitch = R + 8;                                  // 144 / 272 bytes per row
  static constexpr int kWStage = kLsKC * kLsWPitch * 2;
  static constexpr int kAStage = kLsKC * kAPitch * 2;
  static constexpr int kWarpRing = kLsStages * (kWStage + kAStage);
  static constexpr int kRingBytes = 4 * kWarpRing;
  // after the k loop the ring is dead; the reduction buffers live in it
  static constexpr int kRedD = 0;                                        // [4][16][R] fp32
  static constexpr int kRedW = kRedD + 4 * 16 * R * 4;                   // [4][16][32] fp32
  static constexpr int kXchg = kRedW + 4 * 16 * kLsCols * 4;             // rank 0: [8 ranks][16][R + 32] fp32
  static constexpr int kXchgRow = R + kLsCols;
  static constexpr int kD16 = kXchg + 8 * 16 * kXchgRow * 4;             // [16][R + 8] 16 bit
  static constexpr int kSumW = kD16 + 16 * kAPitch * 2;                  // [16][32] fp32: x w summed over the cluster
  static constexpr int kEpilogueBytes = kSumW + 16 * kLsCols * 4;
  // the tile's panel of b, [R][40] 16 bit, is requested when the kernel starts and so lives outside the ring
  static constexpr int kBPanel = kRingBytes > kEpilogueBytes ? kRingBytes : kEpilogueBytes;
  static constexpr int kTotal = kBPanel + R * kLsWPitch * 2;
};

struct LsParams {
  const void* x; const void* w; const void* a; const void* b;
  void* o; void* d;
  int M, N, P;
  int ks;                  // CTAs per cluster = parts of the contraction
};

template <typename T, int R>
__global__ void __launch_bounds__(kLsThreads)
lora_small_kernel(const LsParams p) {
  using SM = LsSmem<R>;
  extern __shared__ __align__(16) uint8_t ls_smem[];
  const uint32_t smem_base = smem_u32(ls_smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t rank = cluster_ctarank();
  const int tile = static_cast<int>(blockIdx.x) / p.ks;
  const int c0 = tile * kLsCols;
  const T* x = static_cast<const T*>(p.x);
  const T* w = static_cast<const T*>(p.w);
  const T* a = static_cast<const T*>(p.a);
  const int k_per_warp = p.N / (4 * p.ks);
  const int k_begin = (static_cast<int>(rank) * 4 + warp) * k_per_warp;
  const int n_chunks = k_per_warp / kLsKC;
  const uint32_t ring = smem_base + warp * SM::kWarpRing;
  auto w_stage = [&](int s) { return ring + s * (SM::kWStage + SM::kAStage); };
  auto a_stage = [&](int s) { return w_stage(s) + SM::kWStage; };

  auto load_stage = [&](int chunk) {
    const int s = chunk % kLsStages;
    const int kk = k_begin + chunk * kLsKC;
#pragma unroll
    for (int i = 0; i < 4; ++i) {                       // w: 32 rows x 4 segments of 8 columns
      const int c = i * 32 + lane, row = c >> 2, seg = c & 3;
      cp_async16(w_stage(s) + row * (kLsWPitch * 2) + seg * 16, w + static_cast<long long>(kk + row) * p.P + c0 + seg * 8);
    }
    constexpr int kSeg = R / 8;
#pragma unroll
    for (int i = 0; i < kSeg; ++i) {                    // a: 32 rows x R/8 segments
      const int c = i * 32 + lane, row = c / kSeg, seg = c % kSeg;
      cp_async16(a_stage(s) + row * (SM::kAPitch * 2) + seg * 16, a + static_cast<long long>(kk + row) * R + seg * 8);
    }
  };

  float acc_w[4][4], acc_d[R / 8][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc_w[i][j] = 0.f;
#pragma unroll
  for (int i = 0; i < R / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc_d[i][j] = 0.f;

  if (rank == 0) {
    // rank 0 alone uses the cluster's panel of b (R rows x 32 columns): asked for now, needed after the k loop
    for (int c = threadIdx.x; c < R * 4; c += kLsThreads) {
      const int row = c >> 2, seg = c & 3;
      cp_async16(smem_base + SM::kBPanel + row * (kLsWPitch * 2) + seg * 16,
                 static_cast<const T*>(p.b) + static_cast<long long>(row) * p.P + c0 + seg * 8);
    }
  }
#pragma unroll
  for (int s = 0; s < kLsStages - 1; ++s) {
    if (s < n_chunks) load_stage(s);
    cp_async_commit();             // the first group also carries rank 0's panel of b
  }
  const bool row_lo = g < p.M, row_hi = g + 8 < p.M;
  const uint32_t* x_lo = reinterpret_cast<const uint32_t*>(x + static_cast<long long>(row_lo ? g : 0) * p.N);
  const uint32_t* x_hi = reinterpret_cast<const uint32_t*>(x + static_cast<long long>(row_hi ? g + 8 : 0) * p.N);
  // x fragments of one chunk (two k steps), fetched one chunk ahead of their use: x comes straight from L2
  uint32_t x_next[kLsKC / 16][4];
  auto load_x = [&](int chunk) {
#pragma unroll
    for (int ks = 0; ks < kLsKC / 16; ++ks) {
      const int k0 = k_begin + chunk * kLsKC + ks * 16;
      x_next[ks][0] = row_lo ? __ldg(x_lo + ((k0 + 2 * t) >> 1)) : 0u;
      x_next[ks][1] = row_hi ? __ldg(x_hi + ((k0 + 2 * t) >> 1)) : 0u;
      x_next[ks][2] = row_lo ? __ldg(x_lo + ((k0 + 8 + 2 * t) >> 1)) : 0u;
      x_next[ks][3] = row_hi ? __ldg(x_hi + ((k0 + 8 + 2 * t) >> 1)) : 0u;
    }
  };
  load_x(0);
  for (int chunk = 0; chunk < n_chunks; ++chunk) {
    uint32_t x_cur[kLsKC / 16][4];
#pragma unroll
    for (int ks = 0; ks < kLsKC / 16; ++ks)
#pragma unroll
      for (int i = 0; i < 4; ++i) x_cur[ks][i] = x_next[ks][i];
    if (chunk + 1 < n_chunks) load_x(chunk + 1);
    cp_async_wait<kLsStages - 2>();
    __syncwarp();
    if (chunk + kLsStages - 1 < n_chunks) load_stage(chunk + kLsStages - 1);
    cp_async_commit();
    const int s = chunk % kLsStages;
#pragma unroll
    for (int ks = 0; ks < kLsKC / 16; ++ks) {
      const uint32_t (&xa)[4] = x_cur[ks];
      const int krow = ks * 16 + (lane & 15);
#pragma unroll
      for (int n2 = 0; n2 < 2; ++n2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(w_stage(s) + krow * (kLsWPitch * 2) + (n2 * 16 + (lane >> 4) * 8) * 2, b0, b1, b2, b3);
        mma16816<T>(acc_w[2 * n2], xa, b0, b1);
        mma16816<T>(acc_w[2 * n2 + 1], xa, b2, b3);
      }
#pragma unroll
      for (int n2 = 0; n2 < R / 16; ++n2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(a_stage(s) + krow * (SM::kAPitch * 2) + (n2 * 16 + (lane >> 4) * 8) * 2, b0, b1, b2, b3);
        mma16816<T>(acc_d[2 * n2], xa, b0, b1);
        mma16816<T>(acc_d[2 * n2 + 1], xa, b2, b3);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();                 // every warp is done with its ring: the reduction buffers take its place

  float* red_d = reinterpret_cast<float*>(ls_smem + SM::kRedD);
  float* red_w = reinterpret_cast<float*>(ls_smem + SM::kRedW);
  T* d16 = reinterpret_cast<T*>(ls_smem + SM::kD16);
#pragma unroll
  for (int n = 0; n < R / 8; ++n) {
    *reinterpret_cast<float2*>(red_d + (warp * 16 + g) * R + n * 8 + 2 * t) = make_float2(acc_d[n][0], acc_d[n][1]);
    *reinterpret_cast<float2*>(red_d + (warp * 16 + g + 8) * R + n * 8 + 2 * t) = make_float2(acc_d[n][2], acc_d[n][3]);
  }
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    *reinterpret_cast<float2*>(red_w + (warp * 16 + g) * kLsCols + n * 8 + 2 * t) = make_float2(acc_w[n][0], acc_w[n][1]);
    *reinterpret_cast<float2*>(red_w + (warp * 16 + g + 8) * kLsCols + n * 8 + 2 * t) = make_float2(acc_w[n][2], acc_w[n][3]);
  }
  __syncthreads();
  // this CTA's part of both sums: its four warps in order, two adjacent columns per item
  constexpr int kDItems = 16 * R / 2 / kLsThreads;
  constexpr int kWItems = 16 * kLsCols / 2 / kLsThreads;
  float2 dsum[kDItems], wsum[kWItems];
#pragma unroll
  for (int j = 0; j < kDItems; ++j) {
    const int i = threadIdx.x + j * kLsThreads, row = i / (R / 2), col = (i % (R / 2)) * 2;
    dsum[j] = *reinterpret_cast<const float2*>(red_d + row * R + col);
#pragma unroll
    for (int ww = 1; ww < 4; ++ww) {
      const float2 v = *reinterpret_cast<const float2*>(red_d + (ww * 16 + row) * R + col);
      dsum[j].x += v.x;
      dsum[j].y += v.y;
    }
  }
#pragma unroll
  for (int j = 0; j < kWItems; ++j) {
    const int i = threadIdx.x + j * kLsThreads, row = i / (kLsCols / 2), col = (i % (kLsCols / 2)) * 2;
    wsum[j] = *reinterpret_cast<const float2*>(red_w + row * kLsCols + col);
#pragma unroll
    for (int ww = 1; ww < 4; ++ww) {
      const float2 v = *reinterpret_cast<const float2*>(red_w + (ww * 16 + row) * kLsCols + col);
      wsum[j].x += v.x;
      wsum[j].y += v.y;
    }
  }
  // every CTA of the cluster is past its ring (its cp.async groups are complete and the values read above are in
  // registers): rank 0's exchange area may be written.  Nothing is published here, so no release fence
  cluster_sync_all_relaxed();
  {
    const uint32_t slot = map_to_rank(smem_base + SM::kXchg, 0) + rank * (16 * SM::kXchgRow * 4);
#pragma unroll
    for (int j = 0; j < kDItems; ++j) {
      const int i = threadIdx.x + j * kLsThreads, row = i / (R / 2), col = (i % (R / 2)) * 2;
      st_cluster_f2(slot + (row * SM::kXchgRow + col) * 4, dsum[j].x, dsum[j].y);
    }
#pragma unroll
    for (int j = 0; j < kWItems; ++j) {
      const int i = threadIdx.x + j * kLsThreads, row = i / (kLsCols / 2), col = (i % (kLsCols / 2)) * 2;
      st_cluster_f2(slot + (row * SM::kXchgRow + R + col) * 4, wsum[j].x, wsum[j].y);
    }
  }
  cluster_sync_all();        // the parts of every rank have landed in rank 0
  if (rank != 0) return;

  // sums over the ranks in order; d rounded to 16 bit (the first cluster stores it)
  const float* xchg = reinterpret_cast<const float*>(ls_smem + SM::kXchg);
  float* sum_w = reinterpret_cast<float*>(ls_smem + SM::kSumW);
#pragma unroll
  for (int j = 0; j < kDItems; ++j) {
    const int i = threadIdx.x + j * kLsThreads, row = i / (R / 2), col = (i % (R / 2)) * 2;
    float2 sum = *reinterpret_cast<const float2*>(xchg + row * SM::kXchgRow + col);
#pragma unroll
    for (int r = 1; r < 8; ++r) {          // independent loads, added in rank order
      if (r < p.ks) {
        const float2 v = *reinterpret_cast<const float2*>(xchg + (r * 16 + row) * SM::kXchgRow + col);
        sum.x += v.x;
        sum.y += v.y;
      }
    }
    const uint32_t packed = Io<T>::pack2(sum.x, sum.y);
    *reinterpret_cast<uint32_t*>(d16 + row * SM::kAPitch + col) = packed;
    if (tile == 0 && row < p.M)
      *reinterpret_cast<uint32_t*>(static_cast<T*>(p.d) + static_cast<long long>(row) * R + col) = packed;
  }
#pragma unroll
  for (int j = 0; j < kWItems; ++j) {
    const int i = threadIdx.x + j * kLsThreads, row = i / (kLsCols / 2), col = (i % (kLsCols / 2)) * 2;
    float2 sum = *reinterpret_cast<const float2*>(xchg + row * SM::kXchgRow + R + col);
#pragma unroll
    for (int r = 1; r < 8; ++r) {
      if (r < p.ks) {
        const float2 v = *reinterpret_cast<const float2*>(xchg + (r * 16 + row) * SM::kXchgRow + R + col);
        sum.x += v.x;
        sum.y += v.y;
      }
    }
    *reinterpret_cast<float2*>(sum_w + row * kLsCols + col) = sum;
  }
  __syncthreads();

  // o columns [8 warp, 8 warp + 8) of this tile: d b on the tensor cores, plus x w
  float acc_o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int ks = 0; ks < R / 16; ++ks) {
    uint32_t da[4];
    da[0] = *reinterpret_cast<const uint32_t*>(d16 + g * SM::kAPitch + ks * 16 + 2 * t);
    da[1] = *reinterpret_cast<const uint32_t*>(d16 + (g + 8) * SM::kAPitch + ks * 16 + 2 * t);
    da[2] = *reinterpret_cast<const uint32_t*>(d16 + g * SM::kAPitch + ks * 16 + 8 + 2 * t);
    da[3] = *reinterpret_cast<const uint32_t*>(d16 + (g + 8) * SM::kAPitch + ks * 16 + 8 + 2 * t);
    uint32_t b0, b1, b2, b3;
    ldmatrix_x4_trans(smem_base + SM::kBPanel + (ks * 16 + (lane & 15)) * (kLsWPitch * 2) +
                          ((warp >> 1) * 16 + (lane >> 4) * 8) * 2,
                      b0, b1, b2, b3);
    if (warp & 1) mma16816<T>(acc_o, da, b2, b3);
    else mma16816<T>(acc_o, da, b0, b1);
  }
  const int col = warp * 8 + 2 * t;
  const float2 xw_lo = *reinterpret_cast<const float2*>(sum_w + g * kLsCols + col);
  const float2 xw_hi = *reinterpret_cast<const float2*>(sum_w + (g + 8) * kLsCols + col);
  T* o = static_cast<T*>(p.o);
  if (row_lo)
    *reinterpret_cast<uint32_t*>(o + static_cast<long long>(g) * p.P + c0 + col) =
        Io<T>::pack2(xw_lo.x + acc_o[0], xw_lo.y + acc_o[1]);
  if (row_hi)
    *reinterpret_cast<uint32_t*>(o + static_cast<long long>(g + 8) * p.P + c0 + col) =
        Io<T>::pack2(xw_hi.x + acc_o[2], xw_hi.y + acc_o[3]);
}

// parts of the contraction (= CTAs per cluster): as many as keep every warp at least one 32-row chunk and the grid
// within one wave of the SMs
int lora_small_parts(const TrnLoraArgs& a, int sm_count) {
  const int tiles = static_cast<int>(a.P / kLsCols);
  int ks = 8;
  while (ks > 1 && ((a.N % (4 * kLsKC * ks)) != 0 || tiles * ks > sm_count)) ks >>= 1;
  return ks;
}

template <typename T, int R>
int launch_small_inst(const TrnLoraArgs& a, cudaStream_t st, const DeviceState& ds) {
  using SM = LsSmem<R>;
  auto kern = lora_small_kernel<T, R>;
  const int rc = ensure_dyn_smem(reinterpret_cast<const void*>(kern), SM::kTotal, ds.device);
  if (rc != TRN_OK) return rc;
  LsParams p{a.x, a.w, a.a, a.b, a.o, a.d, static_cast<int>(a.M), static_cast<int>(a.N), static_cast<int>(a.P),
             lora_small_parts(a, ds.sm_count)};
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(a.P / kLsCols * p.ks), 1, 1);
  cfg.blockDim = dim3(kLsThreads, 1, 1);
  cfg.dynamicSmemBytes = SM::kTotal;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(p.ks);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TRN_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
  return TRN_OK;
}

}  // namespace

bool lora_small_applies(const TrnLoraArgs& a) {
  return a.M <= 16 && (a.N % (4 * kLsKC)) == 0 && (a.P % kLsCols) == 0 && (a.R == 64 || a.R == 128);
}

int launch_lora_small(const TrnLoraArgs& a, cudaStream_t st, const DeviceState& ds) {
  if (a.dtype == TRN_BF16)
    return a.R == 64 ? launch_small_inst<__nv_bfloat16, 64>(a, st, ds) : launch_small_inst<__nv_bfloat16, 128>(a, st, ds);
  if (a.dtype == TRN_FP16)
    return a.R == 64 ? launch_small_inst<__half, 64>(a, st, ds) : launch_small_inst<__half, 128>(a, st, ds);
  return TRN_E_DTYPE;
}

}  // namespace trn
