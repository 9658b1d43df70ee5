// Top-k key selection over per-key scores (KeyFormer / RoCo retention): for every (batch, head) row
// of an fp32 score matrix, the indices of the k largest scores in descending order; equal scores keep
// the lower index first, i.e. torch.sort(descending=True, stable=True)[:k].
// The reference has no kernel for this step (keyformer_llama_benchmark.py only reports C_out).
//
// One CTA per row: scores become 64-bit sort keys (order-preserving bit trick on the float, index in the low word:
// all keys differ, so every correct sort gives the same order) and are sorted with a bitonic network; n <= 8192.
// Thread t holds the E consecutive keys t*E .. t*E+E-1 in registers: compare-exchange strides below E stay inside a
// thread, strides below 32 E go through warp shuffles, and only the strides of 32 E and more — 15 of the 91 stages
// at n = 8192 — go through shared memory with a CTA barrier each (a barrier per stage is what a plain shared-memory
// network pays: 94 us for 142 rows of 8192 against 2x-4x less here).
#include "common.cuh"
#include "host.h"

namespace trn {
namespace {

constexpr int kTopkMaxThreads = 1024;
constexpr int kTopkMaxN = 8192;

// stages j = j_hi, j_hi / 2, ..., 1 (all below 32 E) of the merge phase k2 on the keys in registers
template <int E>
__device__ __forceinline__ void bitonic_low_stages(unsigned long long (&v)[E], int tid, int k2, int j_hi) {
  for (int j = j_hi; j > 0; j >>= 1) {
    if (j >= E) {
      const int lane_mask = j / E;                       // partner thread differs in this bit (within the warp)
      const bool lower = (tid & lane_mask) == 0;
      const bool asc = ((tid * E) & k2) == 0;            // k2 >= 2 j >= 2 E: the direction is the thread's
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const unsigned long long o = __shfl_xor_sync(0xffffffffu, v[e], lane_mask);
        const bool take_min = (lower == asc);
        v[e] = take_min ? (v[e] < o ? v[e] : o) : (v[e] > o ? v[e] : o);
      }
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) {
        if ((e & j) == 0) {
          const int f = e | j;
          const bool asc = (((tid * E) + e) & k2) == 0;
          const unsigned long long a = v[e], b = v[f];
          if ((a > b) == asc) { v[e] = b; v[f] = a; }
        }
      }
    }
  }
}

template <int E>
__global__ void __launch_bounds__(kTopkMaxThreads)
topk_rows_kernel(const float* __restrict__ scores, int32_t* __restrict__ idx_out, int n, int np2, int k,
                 long long row_stride) {
  extern __shared__ unsigned long long keys[];
  const int tid = threadIdx.x, nthreads = blockDim.x;     // nthreads * E == np2
  const float* srow = scores + static_cast<long long>(blockIdx.x) * row_stride;
  unsigned long long v[E];
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const int i = tid * E + e;
    unsigned long long key = ~0ull;
    if (i < n) {
      const float s = srow[i] + 0.0f;                      // -0 -> +0
      uint32_t u = __float_as_uint(s);
      u ^= (u >> 31) ? 0xffffffffu : 0x80000000u;          // ascending unsigned == ascending float
      key = (static_cast<unsigned long long>(~u) << 32) | static_cast<uint32_t>(i);   // descending score
    }
    v[e] = key;
  }
  const int warp_span = 32 * E;                            // keys a warp holds
  // merge phases that fit a warp: registers and shuffles only
  for (int k2 = 2; k2 <= warp_span && k2 <= np2; k2 <<= 1) bitonic_low_stages<E>(v, tid, k2, k2 >> 1);
  // larger phases: the strides of a warp's span and more through shared memory, the rest in registers again
  for (int k2 = 2 * warp_span; k2 <= np2; k2 <<= 1) {
#pragma unroll
    for (int e = 0; e < E; ++e) keys[tid * E + e] = v[e];
    __syncthreads();
    for (int j = k2 >> 1; j >= warp_span; j >>= 1) {
      for (int i = tid; i < np2; i += nthreads) {
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
#pragma unroll
    for (int e = 0; e < E; ++e) v[e] = keys[tid * E + e];
    bitonic_low_stages<E>(v, tid, k2, warp_span >> 1);
    __syncthreads();                                       // the reads above are done before the next phase's stores
  }
  int32_t* orow = idx_out + static_cast<long long>(blockIdx.x) * k;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const int i = tid * E + e;
    if (i < k) orow[i] = static_cast<int32_t>(v[e] & 0xffffffffull);
  }
}

template <int E>
int launch_e(const TrnTopkArgs& a, int np2, cudaStream_t st, const DeviceState& ds) {
  const size_t smem = static_cast<size_t>(np2) * sizeof(unsigned long long);
  int rc = ensure_dyn_smem(reinterpret_cast<const void*>(topk_rows_kernel<E>),
                           kTopkMaxN * static_cast<int>(sizeof(unsigned long long)), ds.device);
  if (rc != TRN_OK) return rc;
  topk_rows_kernel<E><<<static_cast<int>(a.rows), np2 / E, smem, st>>>(a.scores, a.idx_out, a.n, np2, a.k,
                                                                       a.score_row_stride);
  TRN_CUDA_TRY(cudaGetLastError());
  return TRN_OK;
}

}  // namespace

int launch_topk(const TrnTopkArgs& a, cudaStream_t st, const DeviceState& ds) {
  if (a.scores == nullptr || a.idx_out == nullptr) return TRN_E_NULL;
  if (a.rows < 0 || a.n <= 0 || a.n > kTopkMaxN || a.k <= 0 || a.k > a.n) return TRN_E_SHAPE;
  if (a.score_row_stride < a.n || a.rows > 0x7fffffffLL) return TRN_E_SHAPE;
  if (a.rows == 0) return TRN_OK;
  int np2 = 32;                                  // at least one full warp of keys (padding keys sort last)
  while (np2 < a.n) np2 <<= 1;
  // keys per thread: as few as keep the CTA at 1024 threads or less
  if (np2 <= kTopkMaxThreads) return launch_e<1>(a, np2, st, ds);
  if (np2 == 2 * kTopkMaxThreads) return launch_e<2>(a, np2, st, ds);
  if (np2 == 4 * kTopkMaxThreads) return launch_e<4>(a, np2, st, ds);
  return launch_e<8>(a, np2, st, ds);
}

}  // namespace trn
