// Gated MLP for at most 16 tokens (gmlp_benchmark.py:53-74 at the reference's M = 16):
//   o = gate(x w1) * (x w2),  gate(c) = c * sigmoid(c)  or  sigmoid(c).
//
// With 16 rows the operator is a stream of the two weight matrices through the SMs (2 K N 16-bit values, read once)
// and a few microseconds long: latency counts, not the tensor pipe's rate, so — like the small LoRA kernel — this path
// does without tensor memory and TMA descriptors.  A CTA (or a cluster of up to 8 CTAs that split the contraction)
// owns 32 (or, for wide outputs, 64) output columns; warp w of rank r contracts the k range number 4 r + w of BOTH products with warp-level
// mma.m16n8k16 and fp32 accumulators, streaming its [32 x 32] (or [32 x 64]) panels of w1 and w2 through a private cp.async ring (no
// CTA barrier in the loop); x fragments come straight from L2 one chunk ahead.  Partial sums are added in a fixed
// order (the four warps through shared memory, then the ranks through rank 0's shared memory between two cluster
// barriers); rank 0 applies the gate and rounds o once.
#include "common.cuh"
#include "host.h"
#include "small_mma.cuh"

namespace trn {
namespace {

constexpr int kGsThreads = 128;
constexpr int kGsKC = 32;            // k rows per ring stage

// COLS output columns per CTA / cluster: 32 (more CTAs: the shapes whose 32-column tiles fit the SMs in one wave) or
// 64 with a three-stage ring (whole 128-byte lines per row; measured faster once there are more 32-column tiles
// than SMs, e.g. N = 8192: 12.5 against 14.4 us, and slower below that, N = 4096: 6.4 against 5.9 us).
template <int COLS>
struct GsCfg {
  static constexpr int kCols = COLS;
  static constexpr int kStages = (COLS == 32) ? 4 : 3;
  static constexpr int kSeg = COLS / 8;                  // 16-byte segments per staged row
  static constexpr int kNB = COLS / 8;                   // 8-column accumulator blocks per product
  static constexpr int kPitch = COLS + 8;                // +16 bytes per staged row: conflict-free ldmatrix
  static constexpr int kPanel = kGsKC * kPitch * 2;      // one [32 x COLS] panel
  static constexpr int kWarpRing = kStages * 2 * kPanel;
  static constexpr int kRingBytes = 4 * kWarpRing;
  // after the k loop the ring is dead: [4 warps][2 products][16][COLS] fp32, then rank 0's exchange area [8][2][16][COLS]
  static constexpr int kRed = 0;
  static constexpr int kXchg = kRed + 4 * 2 * 16 * COLS * 4;
  static constexpr int kEpilogue = kXchg + 8 * 2 * 16 * COLS * 4;
  static constexpr int kSmem = kRingBytes > kEpilogue ? kRingBytes : kEpilogue;
};

struct GsParams {
  const void* x; const void* w1; const void* w2;
  void* o;
  int M, K, N;
  int ks;                  // CTAs per cluster = parts of the contraction
  int gate;
};

template <typename T, int COLS>
__global__ void __launch_bounds__(kGsThreads)
gmlp_small_kernel(const GsParams p) {
  using Cfg = GsCfg<COLS>;
  constexpr int kGsCols = Cfg::kCols, kGsStages = Cfg::kStages, kGsSeg = Cfg::kSeg, kGsNB = Cfg::kNB;
  constexpr int kGsPitch = Cfg::kPitch, kGsPanel = Cfg::kPanel, kGsWarpRing = Cfg::kWarpRing;
  constexpr int kGsRed = Cfg::kRed, kGsXchg = Cfg::kXchg;
  extern __shared__ __align__(16) uint8_t gs_smem[];
  const uint32_t smem_base = smem_u32(gs_smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t rank = cluster_ctarank();
  const int tile = static_cast<int>(blockIdx.x) / p.ks;
  const int c0 = tile * kGsCols;
  const T* x = static_cast<const T*>(p.x);
  const T* w1 = static_cast<const T*>(p.w1);
  const T* w2 = static_cast<const T*>(p.w2);
  const int k_per_warp = p.K / (4 * p.ks);
  const int k_begin = (static_cast<int>(rank) * 4 + warp) * k_per_warp;
  const int n_chunks = k_per_warp / kGsKC;
  const uint32_t ring = smem_base + warp * kGsWarpRing;
  auto stage1 = [&](int s) { return ring + s * 2 * kGsPanel; };
  auto stage2 = [&](int s) { return stage1(s) + kGsPanel; };

  auto load_stage = [&](int chunk) {
    const int s = chunk % kGsStages;
    const int kk = k_begin + chunk * kGsKC;
#pragma unroll
    for (int i = 0; i < kGsKC * kGsSeg / 32; ++i) {     // kGsKC rows x kGsSeg segments of 8 columns, both matrices
      const int c = i * 32 + lane, row = c / kGsSeg, seg = c % kGsSeg;
      const long long off = static_cast<long long>(kk + row) * p.N + c0 + seg * 8;
      cp_async16(stage1(s) + row * (kGsPitch * 2) + seg * 16, w1 + off);
      cp_async16(stage2(s) + row * (kGsPitch * 2) + seg * 16, w2 + off);
    }
  };

  float acc1[kGsNB][4], acc2[kGsNB][4];
#pragma unroll
  for (int i = 0; i < kGsNB; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc1[i][j] = 0.f; acc2[i][j] = 0.f; }

#pragma unroll
  for (int s = 0; s < kGsStages - 1; ++s) {
    if (s < n_chunks) load_stage(s);
    cp_async_commit();
  }
  const bool row_lo = g < p.M, row_hi = g + 8 < p.M;
  const uint32_t* x_lo = reinterpret_cast<const uint32_t*>(x + static_cast<long long>(row_lo ? g : 0) * p.K);
  const uint32_t* x_hi = reinterpret_cast<const uint32_t*>(x + static_cast<long long>(row_hi ? g + 8 : 0) * p.K);
  uint32_t x_next[kGsKC / 16][4];
  auto load_x = [&](int chunk) {
#pragma unroll
    for (int ks = 0; ks < kGsKC / 16; ++ks) {
      const int k0 = k_begin + chunk * kGsKC + ks * 16;
      x_next[ks][0] = row_lo ? __ldg(x_lo + ((k0 + 2 * t) >> 1)) : 0u;
      x_next[ks][1] = row_hi ? __ldg(x_hi + ((k0 + 2 * t) >> 1)) : 0u;
      x_next[ks][2] = row_lo ? __ldg(x_lo + ((k0 + 8 + 2 * t) >> 1)) : 0u;
      x_next[ks][3] = row_hi ? __ldg(x_hi + ((k0 + 8 + 2 * t) >> 1)) : 0u;
    }
  };
  if (n_chunks > 0) load_x(0);
  for (int chunk = 0; chunk < n_chunks; ++chunk) {
    uint32_t x_cur[kGsKC / 16][4];
#pragma unroll
    for (int ks = 0; ks < kGsKC / 16; ++ks)
#pragma unroll
      for (int i = 0; i < 4; ++i) x_cur[ks][i] = x_next[ks][i];
    if (chunk + 1 < n_chunks) load_x(chunk + 1);
    cp_async_wait<kGsStages - 2>();
    __syncwarp();
    if (chunk + kGsStages - 1 < n_chunks) load_stage(chunk + kGsStages - 1);
    cp_async_commit();
    const int s = chunk % kGsStages;
#pragma unroll
    for (int ks = 0; ks < kGsKC / 16; ++ks) {
      const uint32_t (&xa)[4] = x_cur[ks];
      const int krow = ks * 16 + (lane & 15);
#pragma unroll
      for (int n2 = 0; n2 < kGsNB / 2; ++n2) {
        const uint32_t off = krow * (kGsPitch * 2) + (n2 * 16 + (lane >> 4) * 8) * 2;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(stage1(s) + off, b0, b1, b2, b3);
        mma16816<T>(acc1[2 * n2], xa, b0, b1);
        mma16816<T>(acc1[2 * n2 + 1], xa, b2, b3);
        ldmatrix_x4_trans(stage2(s) + off, b0, b1, b2, b3);
        mma16816<T>(acc2[2 * n2], xa, b0, b1);
        mma16816<T>(acc2[2 * n2 + 1], xa, b2, b3);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();                 // every warp is done with its ring: the reduction buffers take its place

  float* red = reinterpret_cast<float*>(gs_smem + kGsRed);         // [warp][product][16][32]
#pragma unroll
  for (int n = 0; n < kGsNB; ++n) {
    float* r1 = red + ((warp * 2 + 0) * 16) * kGsCols + n * 8 + 2 * t;
    float* r2 = red + ((warp * 2 + 1) * 16) * kGsCols + n * 8 + 2 * t;
    *reinterpret_cast<float2*>(r1 + g * kGsCols) = make_float2(acc1[n][0], acc1[n][1]);
    *reinterpret_cast<float2*>(r1 + (g + 8) * kGsCols) = make_float2(acc1[n][2], acc1[n][3]);
    *reinterpret_cast<float2*>(r2 + g * kGsCols) = make_float2(acc2[n][0], acc2[n][1]);
    *reinterpret_cast<float2*>(r2 + (g + 8) * kGsCols) = make_float2(acc2[n][2], acc2[n][3]);
  }
  __syncthreads();
  // this CTA's part of both sums: its four warps in order; thread = (row, two adjacent columns)
  constexpr int kItems = 16 * kGsCols / 2 / kGsThreads;            // 2 or 4
  float2 s1[kItems], s2[kItems];
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const int i = threadIdx.x + j * kGsThreads, row = i / (kGsCols / 2), col = (i % (kGsCols / 2)) * 2;
    s1[j] = make_float2(0.f, 0.f);
    s2[j] = make_float2(0.f, 0.f);
#pragma unroll
    for (int ww = 0; ww < 4; ++ww) {
      const float2 a = *reinterpret_cast<const float2*>(red + ((ww * 2 + 0) * 16 + row) * kGsCols + col);
      const float2 b = *reinterpret_cast<const float2*>(red + ((ww * 2 + 1) * 16 + row) * kGsCols + col);
      s1[j].x += a.x; s1[j].y += a.y;
      s2[j].x += b.x; s2[j].y += b.y;
    }
  }
  if (p.ks > 1) {
    // every CTA of the cluster is past its ring: rank 0's exchange area may be written (nothing published yet)
    cluster_sync_all_relaxed();
    const uint32_t slot = map_to_rank(smem_base + kGsXchg, 0) + rank * (2 * 16 * kGsCols * 4);
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      const int i = threadIdx.x + j * kGsThreads, row = i / (kGsCols / 2), col = (i % (kGsCols / 2)) * 2;
      st_cluster_f2(slot + (row * kGsCols + col) * 4, s1[j].x, s1[j].y);
      st_cluster_f2(slot + ((16 + row) * kGsCols + col) * 4, s2[j].x, s2[j].y);
    }
    cluster_sync_all();            // the parts of every rank have landed in rank 0
    if (rank != 0) return;
    const float* xchg = reinterpret_cast<const float*>(gs_smem + kGsXchg);
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      const int i = threadIdx.x + j * kGsThreads, row = i / (kGsCols / 2), col = (i % (kGsCols / 2)) * 2;
      s1[j] = make_float2(0.f, 0.f);
      s2[j] = make_float2(0.f, 0.f);
#pragma unroll
      for (int r = 0; r < 8; ++r) {          // independent loads, added in rank order
        if (r < p.ks) {
          const float2 a = *reinterpret_cast<const float2*>(xchg + ((r * 2 + 0) * 16 + row) * kGsCols + col);
          const float2 b = *reinterpret_cast<const float2*>(xchg + ((r * 2 + 1) * 16 + row) * kGsCols + col);
          s1[j].x += a.x; s1[j].y += a.y;
          s2[j].x += b.x; s2[j].y += b.y;
        }
      }
    }
  }
  T* o = static_cast<T*>(p.o);
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const int i = threadIdx.x + j * kGsThreads, row = i / (kGsCols / 2), col = (i % (kGsCols / 2)) * 2;
    if (row < p.M) {
      const float g0 = __fdividef(1.0f, 1.0f + __expf(-s1[j].x)), g1 = __fdividef(1.0f, 1.0f + __expf(-s1[j].y));
      const float a0 = (p.gate == 0 ? s1[j].x * g0 : g0) * s2[j].x;
      const float a1 = (p.gate == 0 ? s1[j].y * g1 : g1) * s2[j].y;
      *reinterpret_cast<uint32_t*>(o + static_cast<long long>(row) * p.N + c0 + col) = Io<T>::pack2(a0, a1);
    }
  }
}

template <int COLS>
int gmlp_small_parts(const TrnGmlpArgs& a, int sm_count) {
  const int tiles = a.N / COLS;
  int ks = 8;
  while (ks > 1 && ((a.K % (4 * kGsKC * ks)) != 0 || tiles * ks > sm_count)) ks >>= 1;
  return ks;
}

template <typename T, int COLS>
int launch_small_inst(const TrnGmlpArgs& a, cudaStream_t st, const DeviceState& ds) {
  using Cfg = GsCfg<COLS>;
  auto kern = gmlp_small_kernel<T, COLS>;
  const int rc = ensure_dyn_smem(reinterpret_cast<const void*>(kern), Cfg::kSmem, ds.device);
  if (rc != TRN_OK) return rc;
  GsParams p{a.x, a.w1, a.w2, a.o, a.M, a.K, a.N, gmlp_small_parts<COLS>(a, ds.sm_count), a.gate};
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(a.N / COLS * p.ks), 1, 1);
  cfg.blockDim = dim3(kGsThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmem;
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

template <typename T>
int launch_small_typed(const TrnGmlpArgs& a, cudaStream_t st, const DeviceState& ds) {
  if ((a.N % 64) == 0 && a.N / 32 > ds.sm_count) return launch_small_inst<T, 64>(a, st, ds);
  return launch_small_inst<T, 32>(a, st, ds);
}

}  // namespace

bool gmlp_small_applies(const TrnGmlpArgs& a) {
  return a.M <= 16 && (a.K % (4 * kGsKC)) == 0 && (a.N % 32) == 0;
}

int launch_gmlp_small(const TrnGmlpArgs& a, cudaStream_t st, const DeviceState& ds) {
  if (a.dtype == TRN_BF16) return launch_small_typed<__nv_bfloat16>(a, st, ds);
  if (a.dtype == TRN_FP16) return launch_small_typed<__half>(a, st, ds);
  return TRN_E_DTYPE;
}

}  // namespace trn
