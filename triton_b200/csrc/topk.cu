// Top-k key selection over per-key scores (KeyFormer / RoCo retention): for every (batch, head) row
// of an fp32 score matrix, the indices of the k largest scores in descending order; equal scores keep
// the lower index first, i.e. torch.sort(descending=True, stable=True)[:k].
// The reference has no kernel for this step (keyformer_llama_benchmark.py only reports C_out).
//
// One CTA per row: scores become 64-bit sort keys (order-preserving bit trick on the float, index in
// the low word) in shared memory and are sorted with a bitonic network; n <= 8192 keys = 64 KiB.
#include "common.cuh"
#include "host.h"

namespace trn {
namespace {

constexpr int kTopkThreads = 1024;
constexpr int kTopkMaxN = 8192;

__global__ void __launch_bounds__(kTopkThreads)
topk_rows_kernel(const float* __restrict__ scores, int32_t* __restrict__ idx_out, int n, int np2, int k,
                 long long row_stride) {
  extern __shared__ unsigned long long keys[];
  const float* srow = scores + static_cast<long long>(blockIdx.x) * row_stride;
  for (int i = threadIdx.x; i < np2; i += kTopkThreads) {
    unsigned long long key = ~0ull;
    if (i < n) {
      const float s = srow[i] + 0.0f;                      // -0 -> +0
      uint32_t u = __float_as_uint(s);
      u ^= (u >> 31) ? 0xffffffffu : 0x80000000u;          // ascending unsigned == ascending float
      key = (static_cast<unsigned long long>(~u) << 32) | static_cast<uint32_t>(i);   // descending score
    }
    keys[i] = key;
  }
  __syncthreads();
  for (int k2 = 2; k2 <= np2; k2 <<= 1) {
    for (int j = k2 >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < np2; i += kTopkThreads) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const bool asc = (i & k2) == 0;
          const unsigned long long a = keys[i], b = keys[ixj];
          if ((a > b) == asc) {
            keys[i] = b;
            keys[ixj] = a;
          }
        }
      }
      __syncthreads();
    }
  }
  int32_t* orow = idx_out + static_cast<long long>(blockIdx.x) * k;
  for (int i = threadIdx.x; i < k; i += kTopkThreads) orow[i] = static_cast<int32_t>(keys[i] & 0xffffffffull);
}

}  // namespace

int launch_topk(const TrnTopkArgs& a, cudaStream_t st, const DeviceState& ds) {
  if (a.scores == nullptr || a.idx_out == nullptr) return TRN_E_NULL;
  if (a.rows < 0 || a.n <= 0 || a.n > kTopkMaxN || a.k <= 0 || a.k > a.n) return TRN_E_SHAPE;
  if (a.score_row_stride < a.n || a.rows > 0x7fffffffLL) return TRN_E_SHAPE;
  if (a.rows == 0) return TRN_OK;
  int np2 = 2;
  while (np2 < a.n) np2 <<= 1;
  const size_t smem = static_cast<size_t>(np2) * sizeof(unsigned long long);
  {
    int rc = ensure_dyn_smem(reinterpret_cast<const void*>(topk_rows_kernel),
                             kTopkMaxN * static_cast<int>(sizeof(unsigned long long)), ds.device);
    if (rc != TRN_OK) return rc;
  }
  topk_rows_kernel<<<static_cast<int>(a.rows), kTopkThreads, smem, st>>>(a.scores, a.idx_out, a.n, np2, a.k,
                                                                         a.score_row_stride);
  TRN_CUDA_TRY(cudaGetLastError());
  return TRN_OK;
}

}  // namespace trn
