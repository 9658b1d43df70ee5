// Diagnostic: how many SM clocks one tcgen05.mma of the shapes used by this library's kernels takes when a
// single thread issues them back to back (one CTA per SM, operands resident in shared / tensor memory).
// The figures are the per-instruction ceiling of the tensor pipe that the GEMM and attention kernels are
// judged against; nothing on the product path calls this.
#include "common.cuh"
#include "host.h"

namespace trn {
namespace {

constexpr int kRateThreads = 320;
constexpr int kRateSmem = 132 * 1024;

// shape: TRN_MMA_* of the header.  traffic != 0: eight more warps stream tcgen05.ld / st over the other
// tensor-memory columns, as the softmax warps of the attention kernel do.
__global__ void __launch_bounds__(kRateThreads, 1)
mma_rate_kernel(int shape, int traffic, int iters, long long* out, int* status) {
  extern __shared__ uint8_t raw[];
  const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
  __shared__ uint64_t bar_mem;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&bar_mem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  Ctl ctl{status, &abort_flag};
  if (warp == 1) {
    if (lane == 0) {
      const bool a_tmem = (shape == TRN_MMA_TS_N128 || shape == TRN_MMA_TS_N64);
      const int n = (shape == TRN_MMA_SS_N64 || shape == TRN_MMA_TS_N64) ? 64 : (shape == TRN_MMA_SS_N256 ? 256 : 128);
      const uint32_t idesc = make_idesc_f16(1, 0, a_tmem ? 1 : 0, 128, n);
      // A: [128 x 128] K-major at base (two 64-column chunks); B: K-major [n x 128] or MN-major [128 x n] after it
      const uint64_t ad = make_smem_desc(base, 0, 1024);
      const uint64_t bd = a_tmem ? make_smem_desc(base + 32768, 16384, 1024) : make_smem_desc(base + 32768, 0, 1024);
      const long long t0 = clock64();
      for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          if (a_tmem) {
            umma_ts(tmem + 256, tmem + kk * 8, bd + static_cast<uint64_t>((kk * 2048) >> 4), idesc, 1u);
          } else {
            const uint64_t off = static_cast<uint64_t>(((kk >> 2) * (n * 128) + (kk & 3) * 32) >> 4);
            const uint64_t aoff = static_cast<uint64_t>(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
            umma_ss(tmem + 256, ad + aoff, bd + off, idesc, 1u);
          }
        }
      }
      umma_commit(bar);
      mbar_wait(bar, 0, ctl, KST_TIMEOUT_MMA);
      const long long t1 = clock64();
      if (blockIdx.x == 0) out[0] = t1 - t0;
    }
    __syncwarp();
  } else if (warp >= 2 && traffic) {
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t col0 = (warp >= 6 ? 128u : 0u);
    uint32_t r[32];
    for (int it = 0; it < iters; ++it) {
      for (int c = 0; c < 4; ++c) {
        tmem_ld32(tmem + lane_addr + col0 + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * 1.0001f);
        tmem_st32(tmem + lane_addr + col0 + c * 32, r);
      }
      tmem_wait_st();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace
}  // namespace trn

using namespace trn;

extern "C" int trinity_probe_mma_rate(int shape, int with_tmem_traffic, int n_mma, double* clocks_per_mma) {
  if (clocks_per_mma == nullptr) return TRN_E_NULL;
  if (shape < TRN_MMA_SS_N64 || shape > TRN_MMA_TS_N64 || n_mma < 8 || n_mma > (1 << 20)) return TRN_E_SHAPE;
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  rc = ensure_dyn_smem(reinterpret_cast<const void*>(mma_rate_kernel), kRateSmem, ds->device);
  if (rc != TRN_OK) return rc;
  long long* out = nullptr;
  TRN_CUDA_TRY(cudaMalloc(&out, sizeof(long long)));
  const int iters = n_mma / 8;
  mma_rate_kernel<<<ds->sm_count, kRateThreads, kRateSmem>>>(shape, with_tmem_traffic, iters, out, ds->status);
  cudaError_t e = cudaDeviceSynchronize();
  long long clk = 0;
  if (e == cudaSuccess) e = cudaMemcpy(&clk, out, sizeof(clk), cudaMemcpyDeviceToHost);
  cudaFree(out);
  if (e != cudaSuccess) return record_cuda_error(e, "trinity_probe_mma_rate");
  *clocks_per_mma = static_cast<double>(clk) / (iters * 8);
  return TRN_OK;
}
